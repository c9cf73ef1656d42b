// Host-side construction of the LLVQ v1 index map: the extended Golay code, the
// equivalence classes of the Leech shells 2..13 in format order, and the flat
// records the device decoders read.
//
// The index format is fixed by the reference and must never drift:
//   - Golay generator 0xC75, codewords sorted by (weight, value)
//     (llvq-core/src/golay.rs:23,62-81);
//   - class enumeration by fixed nested loops (llvq-search/src/classes.rs:144-254),
//     laid out shells ascending, even classes before odd ones
//     (llvq-search/src/index.rs:125-176);
//   - mixed-radix composition inside a class (llvq-search/src/index.rs:26-40).
// Because shells ascend, the cap-12 ball (47-bit index, 301 classes) is a prefix
// of the cap-13 ball (48-bit, 383 classes): one table serves both.
#pragma once
#include <cstdint>
#include <vector>

namespace llvq {

constexpr int kDim = 24;
constexpr int kMaxClasses = 383;
constexpr uint64_t kN13 = 280974212784720ull;  // llvq-core/src/leech.rs:54
constexpr uint64_t kN12 = 111043117458000ull;

// One class, host view. "a" is the only arrangement problem of an odd class (24
// slots) or the on-support problem of an even class (w slots); "b" is the
// off-support problem of an even class (24 - w slots) whose last kind is the
// zero run (value 0, possibly with count 0).
struct ClassInfo {
    int shell = 0;
    bool odd = false;
    int w = 0, p_req = 0, free_n = 0;
    int n_a = 0, n_b = 0;
    uint8_t val_a[8] = {0}, cnt_a[8] = {0};
    uint8_t val_b[4] = {0}, cnt_b[4] = {0};
    uint64_t arr_a = 1, arr_b = 1;  // arrangement counts (multinomials)
    uint64_t offset = 0, card = 0;  // first local index and size, origin excluded
};

// Flat 64-byte record read by the device decoders.
struct alignas(16) DevClass {
    unsigned long long offset;  // idx - 1 - offset = local rank
    unsigned long long arr_a;   // odd: m_arr; even: a_on
    unsigned long long arr_b;   // even: a_off
    unsigned long long cnts_a;  // byte j = count of kind j of problem a
    unsigned int cnts_b;        // byte j = count of kind j of problem b (zero run last)
    unsigned int vals_a;        // nibble j = |value| of kind j of problem a
    unsigned int vals_b;        // nibble j = |value| of kind j of problem b
    float inv_norm;             // 1 / sqrt(16 * shell)
    unsigned short golay_base;  // even: first codeword of weight w; odd: 0
    unsigned char odd, w, p_req, free_n, n_a, n_b;
    unsigned char shell;
    unsigned char pad[7];
};
static_assert(sizeof(DevClass) == 64, "DevClass must stay 64 bytes");

struct Codebook {
    uint32_t golay[4096];
    int bucket[26];                  // bucket[w] = index of the first codeword of weight w
    std::vector<ClassInfo> classes;  // 383, format order
    std::vector<uint64_t> ends;      // offset + card per class
    int n_classes12 = 0;             // 301
    uint64_t total12 = 0, total13 = 0;

    Codebook();
    int class_of(uint64_t i) const;  // i = idx - 1
    void dev_classes(std::vector<DevClass>& out) const;
    // Class search accelerator: for key = (idx - 1) >> shift, the first class whose
    // end exceeds key << shift. Entries: (total13 >> shift) + 2.
    void class_lut(int shift, std::vector<uint16_t>& out) const;
};

// Level table of one class in the canonical order of the reference (descending
// count, ties by descending |value|): ClassLevels, llvq-search/src/fastdec.rs:59-76,401-433.
struct Levels {
    int32_t values[5];
    uint8_t counts[5];
    int len, nonzero;
};
Levels class_levels(const ClassInfo& c);

// The fingerprint recipe of llvq-artifact/src/codebook.rs:129-176, split so that
// the probe points can come from any decoder: `probe_indices` lists, in digest
// order, every index whose decoded point is folded in; `fingerprint_from_points`
// folds the table data and the supplied points (24 int8 each; ok[i] == 0 marks
// an index the decoder refused).
void probe_indices(const Codebook& cb, std::vector<uint64_t>& out);
uint64_t fingerprint_from_points(const Codebook& cb, const std::vector<uint64_t>& idx,
                                 const int8_t* points, const uint8_t* ok);

}  // namespace llvq

namespace llvq {

// Magic division of q < 2^28 by d: q / d == umulhi(q << 4, m) >> s.
void magic28(unsigned int d, unsigned int* m, unsigned int* s);

}  // namespace llvq
