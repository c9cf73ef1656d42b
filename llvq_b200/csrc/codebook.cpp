#include "codebook.h"

#include <algorithm>
#include <cmath>
#include <cstring>

namespace llvq {

namespace {

inline int popc(uint32_t v) { return __builtin_popcount(v); }

uint64_t golay_count(int w) {
    return w == 0 || w == 24 ? 1 : (w == 8 || w == 16) ? 759 : w == 12 ? 2576 : 0;
}

// n! / prod c_j!, accumulated as a product of binomials so that every
// intermediate fits 64 bits (the largest arrangement count of the cap-13 ball is
// 5 354 228 880).
uint64_t arrangements(const uint8_t* cnt, int k) {
    uint64_t total = 1;
    int placed = 0;
    for (int j = 0; j < k; ++j) {
        for (int t = 1; t <= cnt[j]; ++t) {
            // multiply by C(placed + t, t) / C(placed + t - 1, t - 1) = (placed + t) / t
            total = total * (uint64_t)(placed + t) / (uint64_t)t;
        }
        placed += cnt[j];
    }
    return total;
}

struct Seed {  // a class before layout
    int shell;
    bool odd;
    int n[7];  // even: n14,n10,n6,n2,n12,n8,n4 ; odd: n13,n11,n9,n7,n5,n3,n1
};

void enumerate(std::vector<Seed>& even, std::vector<Seed>& odd) {
    const int mx = 16 * 13;
    // Even coset. Word values 14,10,6,2 sit on a Golay codeword of weight w; free
    // values 12,8,4 sit off it. Loop nesting order is part of the format.
    for (int n14 = 0; n14 <= mx / 196; ++n14)
    for (int n10 = 0; n10 <= mx / 100; ++n10)
    for (int n6 = 0; n6 <= mx / 36; ++n6)
    for (int n2 = 0; n2 <= mx / 4; ++n2) {
        const int w = n14 + n10 + n6 + n2;
        if (w > 24 || golay_count(w) == 0) continue;
        const int base = 196 * n14 + 100 * n10 + 36 * n6 + 4 * n2;
        if (base > mx) continue;
        const int room = mx - base;
        for (int n12 = 0; n12 <= room / 144; ++n12)
        for (int n8 = 0; n8 <= room / 64; ++n8)
        for (int n4 = 0; n4 <= room / 16; ++n4) {
            const int norm = base + 144 * n12 + 64 * n8 + 16 * n4;
            if (norm > mx || norm % 16 || w + n12 + n8 + n4 > 24) continue;
            const int m = norm / 16;
            if (m < 2 || m > 13) continue;
            const int s0 = 14 * n14 + 10 * n10 + 6 * n6 + 2 * n2 + 12 * n12 + 8 * n8 + 4 * n4;
            if (w == 0 && ((s0 / 4) & 1)) continue;
            even.push_back(Seed{m, false, {n14, n10, n6, n2, n12, n8, n4}});
        }
    }
    // Odd coset: all 24 coordinates odd; class condition n1 + n7 + n9 odd.
    for (int n13 = 0; n13 <= mx / 169; ++n13)
    for (int n11 = 0; n11 <= mx / 121; ++n11)
    for (int n9 = 0; n9 <= mx / 81; ++n9)
    for (int n7 = 0; n7 <= mx / 49; ++n7)
    for (int n5 = 0; n5 <= mx / 25; ++n5) {
        const int heavy = n13 + n11 + n9 + n7 + n5;
        const int hnorm = 169 * n13 + 121 * n11 + 81 * n9 + 49 * n7 + 25 * n5;
        if (heavy > 24 || hnorm > mx) continue;
        for (int n3 = 0; n3 <= 24 - heavy; ++n3) {
            const int n1 = 24 - heavy - n3;
            const int norm = hnorm + 9 * n3 + n1;
            if (norm > mx || norm % 16) continue;
            const int m = norm / 16;
            if (m < 2 || m > 13) continue;
            if (((n1 + n7 + n9) & 1) == 0) continue;
            odd.push_back(Seed{m, true, {n13, n11, n9, n7, n5, n3, n1}});
        }
    }
}

ClassInfo make_even(const Seed& s) {
    static const int wv[4] = {14, 10, 6, 2};
    static const int fv[3] = {12, 8, 4};
    ClassInfo c;
    c.shell = s.shell;
    c.odd = false;
    int s0 = 0;
    for (int j = 0; j < 4; ++j) {
        if (s.n[j] == 0) continue;
        c.val_a[c.n_a] = (uint8_t)wv[j];
        c.cnt_a[c.n_a] = (uint8_t)s.n[j];
        c.n_a++;
        c.w += s.n[j];
        s0 += wv[j] * s.n[j];
    }
    for (int j = 0; j < 3; ++j) {
        if (s.n[4 + j] == 0) continue;
        c.val_b[c.n_b] = (uint8_t)fv[j];
        c.cnt_b[c.n_b] = (uint8_t)s.n[4 + j];
        c.n_b++;
        c.free_n += s.n[4 + j];
        s0 += fv[j] * s.n[4 + j];
    }
    c.val_b[c.n_b] = 0;  // the zero run is always the last off-support kind
    c.cnt_b[c.n_b] = (uint8_t)(24 - c.w - c.free_n);
    c.n_b++;
    c.p_req = (s0 / 4) & 1;
    c.arr_a = arrangements(c.cnt_a, c.n_a);
    c.arr_b = arrangements(c.cnt_b, c.n_b);
    const uint64_t sign_word = c.w == 0 ? 1ull : 1ull << (c.w - 1);
    c.card = golay_count(c.w) * c.arr_a * c.arr_b * sign_word * (1ull << c.free_n);
    return c;
}

ClassInfo make_odd(const Seed& s) {
    static const int ov[7] = {13, 11, 9, 7, 5, 3, 1};
    ClassInfo c;
    c.shell = s.shell;
    c.odd = true;
    for (int j = 0; j < 7; ++j) {
        if (s.n[j] == 0) continue;
        c.val_a[c.n_a] = (uint8_t)ov[j];
        c.cnt_a[c.n_a] = (uint8_t)s.n[j];
        c.n_a++;
    }
    c.arr_a = arrangements(c.cnt_a, c.n_a);
    c.card = 4096ull * c.arr_a;
    return c;
}

struct Fnv1a {
    uint64_t h = 0xcbf29ce484222325ull;
    void byte(uint8_t b) { h = (h ^ b) * 0x00000100000001b3ull; }
    void u64(uint64_t v) { for (int i = 0; i < 8; ++i) byte((uint8_t)(v >> (8 * i))); }
    void i32(int32_t v) { const uint32_t u = (uint32_t)v; for (int i = 0; i < 4; ++i) byte((uint8_t)(u >> (8 * i))); }
};

uint64_t scramble(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}

// Probe positions of one class, in digest order.
void class_probes(uint64_t lo, uint64_t hi, uint64_t ci, uint64_t out[7]) {
    const uint64_t card = hi - lo + 1;
    for (uint64_t q = 0; q < 4; ++q) out[q] = lo + card * q / 4;
    out[4] = hi;
    for (uint64_t k = 0; k < 2; ++k) out[5 + k] = lo + scramble(ci ^ scramble(k)) % card;
}

}  // namespace

Codebook::Codebook() {
    for (uint32_t m = 0; m < 4096; ++m) {
        uint32_t acc = 0;
        for (int b = 0; b < 12; ++b)
            if ((0xC75u >> b) & 1u) acc ^= m << b;  // m(x) * g(x) over GF(2), degree <= 22
        golay[m] = acc | ((uint32_t)(popc(acc) & 1) << 23);
    }
    std::sort(golay, golay + 4096, [](uint32_t a, uint32_t b) {
        const int wa = popc(a), wb = popc(b);
        return wa != wb ? wa < wb : a < b;
    });
    std::memset(bucket, 0, sizeof bucket);
    for (int i = 0; i < 4096; ++i) bucket[popc(golay[i]) + 1]++;
    for (int w = 0; w < 25; ++w) bucket[w + 1] += bucket[w];

    std::vector<Seed> even, odd;
    enumerate(even, odd);
    uint64_t off = 0;
    for (int m = 2; m <= 13; ++m) {
        for (const Seed& s : even)
            if (s.shell == m) classes.push_back(make_even(s));
        for (const Seed& s : odd)
            if (s.shell == m) classes.push_back(make_odd(s));
        if (m == 12) n_classes12 = (int)classes.size();
    }
    for (ClassInfo& c : classes) {
        c.offset = off;
        off += c.card;
        ends.push_back(off);
    }
    total13 = off;
    total12 = ends[n_classes12 - 1];
}

int Codebook::class_of(uint64_t i) const {
    return (int)(std::upper_bound(ends.begin(), ends.end(), i) - ends.begin());
}

void Codebook::dev_classes(std::vector<DevClass>& out) const {
    out.assign(classes.size(), DevClass{});
    for (size_t ci = 0; ci < classes.size(); ++ci) {
        const ClassInfo& c = classes[ci];
        DevClass& d = out[ci];
        std::memset(&d, 0, sizeof d);
        d.offset = c.offset;
        d.arr_a = c.arr_a;
        d.arr_b = c.arr_b;
        for (int j = 0; j < c.n_a; ++j) {
            d.cnts_a |= (unsigned long long)c.cnt_a[j] << (8 * j);
            d.vals_a |= (unsigned int)c.val_a[j] << (4 * j);
        }
        for (int j = 0; j < c.n_b; ++j) {
            d.cnts_b |= (unsigned int)c.cnt_b[j] << (8 * j);
            d.vals_b |= (unsigned int)c.val_b[j] << (4 * j);
        }
        d.inv_norm = (float)(1.0 / std::sqrt(16.0 * c.shell));
        d.golay_base = c.odd ? 0 : (unsigned short)bucket[c.w];
        d.odd = c.odd;
        d.w = (unsigned char)c.w;
        d.p_req = (unsigned char)c.p_req;
        d.free_n = (unsigned char)c.free_n;
        d.n_a = (unsigned char)c.n_a;
        d.n_b = (unsigned char)c.n_b;
        d.shell = (unsigned char)c.shell;
    }
}

void Codebook::class_lut(int shift, std::vector<uint16_t>& out) const {
    const uint64_t n = (total13 >> shift) + 2;
    out.resize(n);
    for (uint64_t k = 0; k < n; ++k) {
        const uint64_t first = k << shift;
        int ci = first >= total13 ? (int)classes.size() - 1 : class_of(first);
        out[k] = (uint16_t)ci;
    }
}

Levels class_levels(const ClassInfo& c) {
    std::vector<std::pair<int, int>> lv;
    for (int j = 0; j < c.n_a; ++j) lv.push_back({c.val_a[j], c.cnt_a[j]});
    if (!c.odd)
        for (int j = 0; j < c.n_b; ++j)
            if (c.cnt_b[j] > 0) lv.push_back({c.val_b[j], c.cnt_b[j]});
    std::sort(lv.begin(), lv.end(), [](const std::pair<int, int>& a, const std::pair<int, int>& b) {
        return a.second != b.second ? a.second > b.second : a.first > b.first;
    });
    Levels L;
    std::memset(&L, 0, sizeof L);
    L.len = (int)lv.size();
    for (int i = 0; i < L.len && i < 5; ++i) {
        L.values[i] = lv[i].first;
        L.counts[i] = (uint8_t)lv[i].second;
        if (lv[i].first != 0) L.nonzero += lv[i].second;
    }
    return L;
}

void probe_indices(const Codebook& cb, std::vector<uint64_t>& out) {
    out.clear();
    for (size_t ci = 0; ci < cb.classes.size(); ++ci) {
        uint64_t p[7];
        class_probes(cb.classes[ci].offset + 1, cb.ends[ci], ci, p);
        out.insert(out.end(), p, p + 7);
    }
    out.push_back(0);
    out.push_back(kN13 + 1);
}

uint64_t fingerprint_from_points(const Codebook& cb, const std::vector<uint64_t>& idx,
                                 const int8_t* points, const uint8_t* ok) {
    Fnv1a h;
    for (const char* c = "llvq codebook fingerprint v1"; *c; ++c) h.byte((uint8_t)*c);
    h.u64(kDim);
    h.u64(kN13);
    h.u64(0xC75);
    h.u64(4096);
    for (int i = 0; i < 4096; ++i) h.u64(cb.golay[i]);
    h.u64(cb.classes.size());
    size_t q = 0;
    auto fold_probe = [&]() {
        h.u64(idx[q]);
        if (ok[q]) {
            h.byte(1);
            for (int i = 0; i < kDim; ++i) h.i32((int32_t)points[q * kDim + i]);
        } else {
            h.byte(0);
        }
        ++q;
    };
    for (size_t ci = 0; ci < cb.classes.size(); ++ci) {
        const ClassInfo& c = cb.classes[ci];
        h.u64(c.offset + 1);
        h.u64(cb.ends[ci]);
        const Levels L = class_levels(c);
        h.u64((uint64_t)L.len);
        h.u64((uint64_t)L.nonzero);
        h.u64(c.odd ? 1 : 0);
        h.u64((uint64_t)c.shell);
        for (int k = 0; k < 5; ++k) {
            h.i32(L.values[k]);
            h.byte(L.counts[k]);
        }
        for (int k = 0; k < 7; ++k) fold_probe();
    }
    fold_probe();
    fold_probe();
    return h.h;
}

}  // namespace llvq

// ---------------------------------------------------------------------------
// Magic division (tables of the even-coset decoder)
// ---------------------------------------------------------------------------

namespace llvq {

void magic28(unsigned int d, unsigned int* m, unsigned int* s) {
    unsigned int l = 0;
    while ((1u << l) < d) ++l;  // ceil(log2 d)
    const unsigned long long pow = 1ull << (28 + l);
    *m = (unsigned int)((pow + d - 1) / d);  // ceil(2^(28+l) / d) <= 2^29 + 1
    *s = l;
}

}  // namespace llvq
