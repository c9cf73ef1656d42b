// CPU oracle for the LLVQ archive-code dequant-GEMV path.
//
// TEST INFRASTRUCTURE ONLY. This file restates, on the CPU, the algorithm the
// reference (pjmalandrino/llvq) runs for this path. Nothing in the shipped
// library links, loads or calls it; only the parity tests, the smoke check and
// the CPU-baseline leg of the benchmark do, and only as the checker.
//
// Parity status: PINNED. The restatement reproduces the reference's published
// codebook fingerprint 0x338f420f11866319
// (llvq-artifact/tests/codebook_fingerprint.rs:58), which digests the Golay
// table, every class range and level table and ~7 decoded probe points in each
// of the 383 classes, plus N(13) (llvq-core/src/leech.rs:54) and the
// reference's packing known-answer vectors (llvq-search/tests/g6_pack.rs).
//
// What follows which reference file:
//   Golay code ............ llvq-core/src/golay.rs:62-81
//   Leech membership ...... llvq-core/src/leech.rs:76-101,132-141
//   class enumeration ..... llvq-search/src/classes.rs:144-254
//   class layout .......... llvq-search/src/index.rs:120-181
//   decode (u128 form) .... llvq-search/src/index.rs:101-118,334-435
//   decode (u64 form) ..... llvq-search/src/fastdec.rs:173-194,321-399
//   encode ................ llvq-search/src/index.rs:190-330
//   level tables .......... llvq-search/src/fastdec.rs:401-433
//   fingerprint ........... llvq-artifact/src/codebook.rs:56-176
//   bit packing ........... llvq-search/src/pack.rs:113-137,
//                           llvq-artifact/src/format.rs:185-200,362-368
//   reconstruct ........... llvq-quant/src/quantizer.rs:354-367
//   dense decode .......... llvq-artifact/src/format.rs:416-439
//   f64 reference rows .... llvq-cuda/src/bin/matvec.rs:284-316
//
// Build: g++ -O3 -march=x86-64-v3 -std=c++17 -shared -fPIC -pthread

#include <algorithm>
#include <array>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

namespace {

typedef unsigned __int128 u128;
constexpr int DIM = 24;
constexpr uint64_t N13 = 280974212784720ull;  // llvq-core/src/leech.rs:54

// ---------------------------------------------------------------- Golay ----

struct GolayCode {
    std::vector<uint32_t> flat;  // weight-major, ascending inside a weight
    int offsets[26];

    GolayCode() {
        flat.resize(4096);
        for (uint32_t m = 0; m < 4096; ++m) {
            // carry-less product m(x) * g2(x), g2 = 0xC75 (golay.rs:23,62-70)
            uint32_t acc = 0, a = m, b = 0xC75u;
            while (b) {
                if (b & 1u) acc ^= a;
                a <<= 1;
                b >>= 1;
            }
            uint32_t parity = (uint32_t)__builtin_popcount(acc) & 1u;
            flat[m] = acc | (parity << 23);
        }
        std::sort(flat.begin(), flat.end(), [](uint32_t x, uint32_t y) {
            int wx = __builtin_popcount(x), wy = __builtin_popcount(y);
            return wx != wy ? wx < wy : x < y;
        });
        std::fill(offsets, offsets + 26, 0);
        for (uint32_t c : flat) offsets[__builtin_popcount(c) + 1]++;
        for (int w = 0; w < 25; ++w) offsets[w + 1] += offsets[w];
    }
    const uint32_t* bucket(int w, int* len) const {
        *len = offsets[w + 1] - offsets[w];
        return flat.data() + offsets[w];
    }
    int rank_in_weight(uint32_t word) const {
        int w = __builtin_popcount(word);
        if (w > 24) return -1;
        int len;
        const uint32_t* b = bucket(w, &len);
        const uint32_t* p = std::lower_bound(b, b + len, word);
        return (p != b + len && *p == word) ? (int)(p - b) : -1;
    }
    int rank(uint32_t word) const {
        int r = rank_in_weight(word);
        return r < 0 ? -1 : offsets[__builtin_popcount(word)] + r;
    }
    bool contains(uint32_t word) const { return rank_in_weight(word) >= 0; }
};

uint64_t gamma_w(int w) {
    switch (w) {
        case 0: return 1;
        case 8: return 759;
        case 12: return 2576;
        case 16: return 759;
        case 24: return 1;
        default: return 0;
    }
}

// -------------------------------------------------------------- classes ----

struct Class {
    int shell = 0;
    bool odd = false;
    // even side
    int w = 0, p_req = 0;
    std::vector<std::pair<int, int>> word, free_;  // (value, count), descending
    std::vector<int> off_counts;                   // free kinds then the zero run
    u128 a_on = 0, a_off = 0, s_w = 0, s_f = 0;
    // odd side
    std::vector<std::pair<int, int>> vals;
    u128 m_arr = 0;
    uint64_t offset = 0, card = 0;
};

u128 factorial(int n) {
    u128 f = 1;
    for (int i = 2; i <= n; ++i) f *= (u128)i;
    return f;
}

u128 multinomial(const int* counts, int k) {
    int n = 0;
    for (int i = 0; i < k; ++i) n += counts[i];
    u128 m = factorial(n);
    for (int i = 0; i < k; ++i) m /= factorial(counts[i]);
    return m;
}

struct RawClasses {
    std::vector<Class> even, odd;
};

// classes.rs:144-254 — the nested-loop order is part of the index format.
RawClasses enumerate_classes(int max_shell) {
    RawClasses out;
    const int mx = 16 * max_shell;
    for (int n14 = 0; n14 <= mx / 196; ++n14)
    for (int n10 = 0; n10 <= mx / 100; ++n10)
    for (int n6 = 0; n6 <= mx / 36; ++n6)
    for (int n2 = 0; n2 <= mx / 4; ++n2) {
        int w = n14 + n10 + n6 + n2;
        if (w > 24 || gamma_w(w) == 0) continue;
        int base = 196 * n14 + 100 * n10 + 36 * n6 + 4 * n2;
        if (base > mx) continue;
        for (int n12 = 0; n12 <= (mx - base) / 144; ++n12)
        for (int n8 = 0; n8 <= (mx - base) / 64; ++n8)
        for (int n4 = 0; n4 <= (mx - base) / 16; ++n4) {
            int norm = base + 144 * n12 + 64 * n8 + 16 * n4;
            int total = w + n12 + n8 + n4;
            if (norm > mx || total > 24 || norm % 16 != 0) continue;
            int m = norm / 16;
            if (m < 2 || m > max_shell) continue;
            int s0 = 2 * n2 + 6 * n6 + 10 * n10 + 14 * n14 + 4 * n4 + 8 * n8 + 12 * n12;
            int p_req = (s0 / 4) % 2;
            if (w == 0 && p_req != 0) continue;
            Class c;
            c.shell = m;
            c.w = w;
            c.p_req = p_req;
            const int wv[4][2] = {{14, n14}, {10, n10}, {6, n6}, {2, n2}};
            for (auto& e : wv) if (e[1] > 0) c.word.push_back({e[0], e[1]});
            const int fv[3][2] = {{12, n12}, {8, n8}, {4, n4}};
            for (auto& e : fv) if (e[1] > 0) c.free_.push_back({e[0], e[1]});
            out.even.push_back(c);
        }
    }
    for (int n13 = 0; n13 <= mx / 169; ++n13)
    for (int n11 = 0; n11 <= mx / 121; ++n11)
    for (int n9 = 0; n9 <= mx / 81; ++n9)
    for (int n7 = 0; n7 <= mx / 49; ++n7)
    for (int n5 = 0; n5 <= mx / 25; ++n5) {
        int heavy = n13 + n11 + n9 + n7 + n5;
        if (heavy > 24) continue;
        int hnorm = 169 * n13 + 121 * n11 + 81 * n9 + 49 * n7 + 25 * n5;
        if (hnorm > mx) continue;
        for (int n3 = 0; n3 <= 24 - heavy; ++n3) {
            int n1 = 24 - heavy - n3;
            int norm = hnorm + 9 * n3 + n1;
            if (norm > mx || norm % 16 != 0) continue;
            int m = norm / 16;
            if (m < 2 || m > max_shell) continue;
            if ((n1 + n7 + n9) % 2 != 1) continue;
            Class c;
            c.shell = m;
            c.odd = true;
            const int ov[7][2] = {{13, n13}, {11, n11}, {9, n9}, {7, n7}, {5, n5}, {3, n3}, {1, n1}};
            for (auto& e : ov) if (e[1] > 0) c.vals.push_back({e[0], e[1]});
            out.odd.push_back(c);
        }
    }
    return out;
}

// ClassLevels of fastdec.rs:401-433: descending count, ties by descending value.
struct Levels {
    int values[5] = {0, 0, 0, 0, 0};
    int counts[5] = {0, 0, 0, 0, 0};
    int len = 0, nonzero = 0;
};

struct Codebook {
    GolayCode golay;
    std::vector<Class> classes;   // format order for the ball of `cap`
    std::vector<uint64_t> ends;   // offset + card
    std::vector<Levels> levels;
    uint64_t total = 0;
    int cap;

    explicit Codebook(int cap_) : cap(cap_) {
        RawClasses rc = enumerate_classes(cap);
        // index.rs:125-176: shells ascending, even classes then odd classes.
        for (int m = 2; m <= cap; ++m) {
            for (const Class& e : rc.even) {
                if (e.shell != m) continue;
                Class c = e;
                int free_n = 0;
                for (auto& f : c.free_) free_n += f.second;
                int n0 = 24 - c.w - free_n;
                for (auto& f : c.free_) c.off_counts.push_back(f.second);
                c.off_counts.push_back(n0);
                std::vector<int> wc;
                for (auto& f : c.word) wc.push_back(f.second);
                c.a_on = multinomial(wc.data(), (int)wc.size());
                c.a_off = multinomial(c.off_counts.data(), (int)c.off_counts.size());
                c.s_w = c.w == 0 ? (u128)1 : ((u128)1 << (c.w - 1));
                c.s_f = (u128)1 << free_n;
                c.card = (uint64_t)((u128)gamma_w(c.w) * c.a_on * c.a_off * c.s_w * c.s_f);
                classes.push_back(c);
                std::vector<std::pair<int, int>> lv(c.word);
                lv.insert(lv.end(), c.free_.begin(), c.free_.end());
                if (n0 > 0) lv.push_back({0, n0});
                levels.push_back(make_levels(lv));
            }
            for (const Class& o : rc.odd) {
                if (o.shell != m) continue;
                Class c = o;
                std::vector<int> cs;
                for (auto& f : c.vals) cs.push_back(f.second);
                c.m_arr = multinomial(cs.data(), (int)cs.size());
                c.card = (uint64_t)(4096 * c.m_arr);
                classes.push_back(c);
                levels.push_back(make_levels(c.vals));
            }
        }
        uint64_t off = 0;
        for (Class& c : classes) {
            c.offset = off;
            off += c.card;
            ends.push_back(off);
        }
        total = off;
    }

    static Levels make_levels(std::vector<std::pair<int, int>> lv) {
        std::sort(lv.begin(), lv.end(), [](const std::pair<int, int>& a, const std::pair<int, int>& b) {
            return a.second != b.second ? a.second > b.second : a.first > b.first;
        });
        Levels L;
        L.len = (int)lv.size();
        for (int i = 0; i < L.len && i < 5; ++i) {
            L.values[i] = lv[i].first;
            L.counts[i] = lv[i].second;
            if (lv[i].first != 0) L.nonzero += lv[i].second;
        }
        return L;
    }

    int class_of(uint64_t i) const {  // i = idx - 1
        return (int)(std::upper_bound(ends.begin(), ends.end(), i) - ends.begin());
    }

    // ---- decode, u128 form (index.rs:101-118,334-435) ----
    static void perm_unrank(u128 rank, int* counts, int k, int* out, int n_slots) {
        for (int s = 0; s < n_slots; ++s) {
            for (int j = 0; j < k; ++j) {
                if (counts[j] == 0) continue;
                counts[j]--;
                u128 m = multinomial(counts, k);
                if (rank < m) {
                    out[s] = j;
                    break;
                }
                rank -= m;
                counts[j]++;
            }
        }
    }

    bool decode_ref(uint64_t idx, int32_t* p) const {
        std::fill(p, p + DIM, 0);
        if (idx == 0) return true;
        uint64_t i = idx - 1;
        if (i >= total) return false;
        const Class& c = classes[class_of(i)];
        u128 local = (u128)(i - c.offset);
        if (!c.odd) {
            u128 r_sf = local % c.s_f; local /= c.s_f;
            u128 r_sw = local % c.s_w; local /= c.s_w;
            u128 r_off = local % c.a_off; local /= c.a_off;
            u128 r_on = local % c.a_on;
            int g = (int)(local / c.a_on);
            int blen;
            uint32_t cw = golay.bucket(c.w, &blen)[g];
            int wc[4] = {0, 0, 0, 0};
            for (size_t t = 0; t < c.word.size(); ++t) wc[t] = c.word[t].second;
            int on_kinds[DIM] = {0};
            perm_unrank(r_on, wc, (int)c.word.size(), on_kinds, c.w);
            int sign[DIM] = {0};
            int par = 0;
            for (int j = 0; j + 1 < c.w; ++j) {
                int b = (int)((r_sw >> j) & 1);
                sign[j] = b;
                par ^= b;
            }
            if (c.w > 0) sign[c.w - 1] = par ^ c.p_req;
            int slot = 0;
            for (int k = 0; k < DIM; ++k) {
                if ((cw >> k) & 1u) {
                    int v = c.word[on_kinds[slot]].first;
                    p[k] = sign[slot] ? -v : v;
                    slot++;
                }
            }
            int oc[8] = {0};
            int n_off = (int)c.off_counts.size();
            for (int t = 0; t < n_off; ++t) oc[t] = c.off_counts[t];
            int off_kinds[DIM] = {0};
            perm_unrank(r_off, oc, n_off, off_kinds, DIM - c.w);
            int zero_kind = (int)c.free_.size();
            slot = 0;
            int fbit = 0;
            for (int k = 0; k < DIM; ++k) {
                if (!((cw >> k) & 1u)) {
                    int kd = off_kinds[slot];
                    if (kd != zero_kind) {
                        int v = c.free_[kd].first;
                        p[k] = ((r_sf >> fbit) & 1) ? -v : v;
                        fbit++;
                    }
                    slot++;
                }
            }
        } else {
            u128 r_arr = local % c.m_arr;
            int g = (int)(local / c.m_arr);
            uint32_t cw = golay.flat[g];
            int cs[8] = {0};
            int k = (int)c.vals.size();
            for (int t = 0; t < k; ++t) cs[t] = c.vals[t].second;
            int kinds[DIM] = {0};
            perm_unrank(r_arr, cs, k, kinds, DIM);
            for (int q = 0; q < DIM; ++q) {
                int v = c.vals[kinds[q]].first;
                int a = (v % 4 == 3) ? v : -v;
                p[q] = ((cw >> q) & 1u) ? a : -a;
            }
        }
        return true;
    }

    // ---- decode, u64 form with M' = M*c/n (fastdec.rs:173-194,321-399) ----
    static void unrank_fast(uint64_t rank, int* counts, int k, uint64_t m0, int* out, int n_slots) {
        uint64_t m = m0;
        uint64_t n = (uint64_t)n_slots;
        for (int s = 0; s < n_slots; ++s) {
            for (int j = 0; j < k; ++j) {
                uint64_t c = (uint64_t)counts[j];
                if (c == 0) continue;
                uint64_t mj = m * c / n;
                if (rank < mj) {
                    out[s] = j;
                    counts[j]--;
                    m = mj;
                    break;
                }
                rank -= mj;
            }
            n--;
        }
    }

    bool decode_fast(uint64_t idx, int32_t* p) const {
        std::fill(p, p + DIM, 0);
        if (idx == 0) return true;
        uint64_t i = idx - 1;
        if (i >= total) return false;
        const Class& c = classes[class_of(i)];
        uint64_t local = i - c.offset;
        if (c.odd) {
            uint64_t m_arr = (uint64_t)c.m_arr;
            uint64_t r_arr = local % m_arr;
            uint32_t cw = golay.flat[local / m_arr];
            int cs[8] = {0};
            int k = (int)c.vals.size();
            for (int t = 0; t < k; ++t) cs[t] = c.vals[t].second;
            int kinds[DIM] = {0};
            unrank_fast(r_arr, cs, k, m_arr, kinds, DIM);
            for (int q = 0; q < DIM; ++q) {
                int v = c.vals[kinds[q]].first;
                int a = (v % 4 == 3) ? v : -v;
                p[q] = ((cw >> q) & 1u) ? a : -a;
            }
        } else {
            uint64_t s_f = (uint64_t)c.s_f, s_w = (uint64_t)c.s_w;
            uint64_t a_off = (uint64_t)c.a_off, a_on = (uint64_t)c.a_on;
            uint64_t r_sf = local % s_f; local /= s_f;
            uint64_t r_sw = local % s_w; local /= s_w;
            uint64_t r_off = local % a_off; local /= a_off;
            uint64_t r_on = local % a_on;
            int blen;
            uint32_t cw = golay.bucket(c.w, &blen)[local / a_on];
            int wc[8] = {0};
            for (size_t t = 0; t < c.word.size(); ++t) wc[t] = c.word[t].second;
            int on_kinds[DIM] = {0};
            unrank_fast(r_on, wc, (int)c.word.size(), a_on, on_kinds, c.w);
            int oc[8] = {0};
            int n_off = (int)c.off_counts.size();
            for (int t = 0; t < n_off; ++t) oc[t] = c.off_counts[t];
            int off_kinds[DIM] = {0};
            unrank_fast(r_off, oc, n_off, a_off, off_kinds, DIM - c.w);
            int sign[DIM] = {0};
            int par = 0;
            for (int j = 0; j + 1 < c.w; ++j) {
                int b = (int)((r_sw >> j) & 1);
                sign[j] = b;
                par ^= b;
            }
            if (c.w > 0) sign[c.w - 1] = par ^ c.p_req;
            int zero_kind = n_off - 1;
            int s_on = 0, s_off = 0, fbit = 0;
            for (int q = 0; q < DIM; ++q) {
                if ((cw >> q) & 1u) {
                    int v = c.word[on_kinds[s_on]].first;
                    p[q] = sign[s_on] ? -v : v;
                    s_on++;
                } else {
                    int kd = off_kinds[s_off];
                    if (kd != zero_kind) {
                        int v = c.free_[kd].first;
                        p[q] = ((r_sf >> fbit) & 1) ? -v : v;
                        fbit++;
                    }
                    s_off++;
                }
            }
        }
        return true;
    }

    // ---- membership and encode (leech.rs:76-101; index.rs:190-330) ----
    bool contains(const int32_t* x) const {
        int par = ((x[0] % 2) + 2) % 2;
        for (int i = 0; i < DIM; ++i)
            if ((((x[i] % 2) + 2) % 2) != par) return false;
        uint32_t word = 0;
        for (int i = 0; i < DIM; ++i) {
            int h = (x[i] - par) >> 1;
            if ((((h % 2) + 2) % 2) == 1) word |= 1u << i;
        }
        if (!golay.contains(word)) return false;
        long s = 0;
        for (int i = 0; i < DIM; ++i) s += x[i];
        return (((s % 8) + 8) % 8) == 4 * par;
    }

    static u128 perm_rank(const int* kind_at, int n_slots, int* counts, int k) {
        u128 rank = 0;
        for (int s = 0; s < n_slots; ++s) {
            int kd = kind_at[s];
            for (int j = 0; j < kd; ++j) {
                if (counts[j] > 0) {
                    counts[j]--;
                    rank += multinomial(counts, k);
                    counts[j]++;
                }
            }
            counts[kd]--;
        }
        return rank;
    }

    // returns 1 and the index, or 0 when x is outside the ball
    int encode(const int32_t* x, uint64_t* out) const {
        bool zero = true;
        for (int i = 0; i < DIM; ++i) zero = zero && x[i] == 0;
        if (zero) { *out = 0; return 1; }
        if (!contains(x)) return 0;
        long n2 = 0;
        for (int i = 0; i < DIM; ++i) n2 += (long)x[i] * x[i];
        if (n2 % 16) return 0;
        int m = (int)(n2 / 16);
        if (m < 2 || m > cap) return 0;
        int par = ((x[0] % 2) + 2) % 2;
        uint32_t cw = 0;
        for (int i = 0; i < DIM; ++i) {
            int h = (x[i] - par) >> 1;
            if ((((h % 2) + 2) % 2) == 1) cw |= 1u << i;
        }
        int by_val[16] = {0};
        for (int i = 0; i < DIM; ++i) by_val[std::abs(x[i])]++;
        for (const Class& c : classes) {
            if (c.shell != m || c.odd != (par == 1)) continue;
            int sig[16] = {0};
            if (c.odd) {
                for (auto& f : c.vals) sig[f.first] = f.second;
            } else {
                for (auto& f : c.word) sig[f.first] = f.second;
                for (auto& f : c.free_) sig[f.first] = f.second;
                sig[0] = by_val[0];
            }
            if (std::memcmp(sig, by_val, sizeof sig) != 0) continue;
            if (c.odd) {
                int g = golay.rank(cw);
                if (g < 0) return 0;
                int kinds[DIM];
                for (int i = 0; i < DIM; ++i) {
                    int av = std::abs(x[i]);
                    int kd = -1;
                    for (size_t t = 0; t < c.vals.size(); ++t) if (c.vals[t].first == av) kd = (int)t;
                    if (kd < 0) return 0;
                    kinds[i] = kd;
                }
                int cs[8] = {0};
                int k = (int)c.vals.size();
                for (int t = 0; t < k; ++t) cs[t] = c.vals[t].second;
                u128 r_arr = perm_rank(kinds, DIM, cs, k);
                *out = 1 + c.offset + (uint64_t)((u128)g * c.m_arr + r_arr);
                return 1;
            }
            int g = golay.rank_in_weight(cw);
            if (g < 0) return 0;
            int on_kinds[DIM], n_on = 0, sign_bits[DIM];
            for (int i = 0; i < DIM; ++i) {
                if ((cw >> i) & 1u) {
                    int av = std::abs(x[i]);
                    int kd = -1;
                    for (size_t t = 0; t < c.word.size(); ++t) if (c.word[t].first == av) kd = (int)t;
                    if (kd < 0) return 0;
                    on_kinds[n_on] = kd;
                    sign_bits[n_on] = x[i] < 0;
                    n_on++;
                }
            }
            int wc[4] = {0, 0, 0, 0};
            for (size_t t = 0; t < c.word.size(); ++t) wc[t] = c.word[t].second;
            u128 r_on = perm_rank(on_kinds, n_on, wc, (int)c.word.size());
            u128 r_sw = 0;
            for (int j = 0; j + 1 < c.w; ++j) r_sw |= (u128)sign_bits[j] << j;
            int zero_kind = (int)c.free_.size();
            int off_kinds[DIM], n_offs = 0, nfb = 0;
            u128 r_sf = 0;
            for (int i = 0; i < DIM; ++i) {
                if (!((cw >> i) & 1u)) {
                    if (x[i] == 0) {
                        off_kinds[n_offs++] = zero_kind;
                    } else {
                        int av = std::abs(x[i]);
                        int kd = -1;
                        for (size_t t = 0; t < c.free_.size(); ++t) if (c.free_[t].first == av) kd = (int)t;
                        if (kd < 0) return 0;
                        off_kinds[n_offs++] = kd;
                        r_sf |= (u128)(x[i] < 0) << nfb;
                        nfb++;
                    }
                }
            }
            int oc[8] = {0};
            int n_off = (int)c.off_counts.size();
            for (int t = 0; t < n_off; ++t) oc[t] = c.off_counts[t];
            u128 r_off = perm_rank(off_kinds, n_offs, oc, n_off);
            u128 local = ((((u128)g * c.a_on + r_on) * c.a_off + r_off) * c.s_w + r_sw) * c.s_f + r_sf;
            *out = 1 + c.offset + (uint64_t)local;
            return 1;
        }
        return 0;
    }
};

const Codebook& book13() {
    static Codebook b(13);
    return b;
}
const Codebook& book12() {
    static Codebook b(12);
    return b;
}
const Codebook& book(int cap) { return cap == 13 ? book13() : book12(); }

// ---------------------------------------------------------- fingerprint ----

struct Fnv {
    uint64_t h = 0xcbf29ce484222325ull;
    void byte(uint8_t b) { h ^= b; h *= 0x00000100000001b3ull; }
    void u64(uint64_t v) { for (int i = 0; i < 8; ++i) byte((uint8_t)(v >> (8 * i))); }
    void i32(int32_t v) { uint32_t u = (uint32_t)v; for (int i = 0; i < 4; ++i) byte((uint8_t)(u >> (8 * i))); }
};

uint64_t mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}

void probe(Fnv& h, const Codebook& cb, uint64_t idx) {
    h.u64(idx);
    int32_t p[DIM];
    if (cb.decode_ref(idx, p)) {
        h.byte(1);
        for (int i = 0; i < DIM; ++i) h.i32(p[i]);
    } else {
        h.byte(0);
    }
}

uint64_t fingerprint() {  // codebook.rs:129-176
    const Codebook& cb = book13();
    Fnv h;
    const char* dom = "llvq codebook fingerprint v1";
    for (const char* c = dom; *c; ++c) h.byte((uint8_t)*c);
    h.u64(DIM);
    h.u64(N13);
    h.u64(0xC75);
    h.u64(cb.golay.flat.size());
    for (uint32_t w : cb.golay.flat) h.u64(w);
    h.u64(cb.classes.size());
    for (size_t ci = 0; ci < cb.classes.size(); ++ci) {
        uint64_t lo = cb.classes[ci].offset + 1, hi = cb.ends[ci];
        h.u64(lo);
        h.u64(hi);
        const Levels& lv = cb.levels[ci];
        h.u64((uint64_t)lv.len);
        h.u64((uint64_t)lv.nonzero);
        h.u64(cb.classes[ci].odd ? 1 : 0);
        h.u64((uint64_t)cb.classes[ci].shell);
        for (int k = 0; k < 5; ++k) {
            h.i32(lv.values[k]);
            h.byte((uint8_t)lv.counts[k]);
        }
        uint64_t card = hi - lo + 1;
        for (uint64_t num = 0; num < 4; ++num) probe(h, cb, lo + card * num / 4);
        probe(h, cb, hi);
        for (uint64_t k = 0; k < 2; ++k) probe(h, cb, lo + mix64((uint64_t)ci ^ mix64(k)) % card);
    }
    probe(h, cb, 0);
    probe(h, cb, N13 + 1);
    return h.h;
}

// read the 48-bit big-endian record of block b (pack.rs:113-137; format.rs:362-368)
inline uint64_t read_code48(const uint8_t* codes, size_t b) {
    const uint8_t* p = codes + 6 * b;
    uint64_t v = 0;
    for (int i = 0; i < 6; ++i) v = (v << 8) | p[i];
    return v;
}

inline int shell_of(const int32_t* p) {
    long n2 = 0;
    for (int i = 0; i < DIM; ++i) n2 += (long)p[i] * p[i];
    return (int)(n2 / 16);
}

template <class F>
void parallel_rows(int64_t n, int threads, F f) {
    if (threads <= 1 || n < 2) { f(0, n); return; }
    std::vector<std::thread> th;
    int64_t chunk = (n + threads - 1) / threads;
    for (int t = 0; t < threads; ++t) {
        int64_t lo = t * chunk, hi = std::min(n, lo + chunk);
        if (lo >= hi) break;
        th.emplace_back([=] { f(lo, hi); });
    }
    for (auto& t : th) t.join();
}

}  // namespace

extern "C" {

uint64_t oracle_fingerprint(void) { return fingerprint(); }

uint64_t oracle_ball_size(int cap) { return book(cap).total; }
int oracle_n_classes(int cap) { return (int)book(cap).classes.size(); }

// Generic MSB-first bit writer/reader of pack.rs, for the packing known answers.
// Writes `n` values of `width` bits; returns the number of bytes produced.
int64_t oracle_pack_bits(const uint64_t* vals, int64_t n, int width, uint8_t* out, int64_t cap_bytes) {
    int64_t bitpos = 0;
    int64_t need = (n * width + 7) / 8;
    if (need > cap_bytes) return -1;
    std::memset(out, 0, (size_t)need);
    for (int64_t i = 0; i < n; ++i)
        for (int b = width - 1; b >= 0; --b) {
            if ((vals[i] >> b) & 1) out[bitpos >> 3] |= (uint8_t)(0x80u >> (bitpos & 7));
            bitpos++;
        }
    return need;
}
void oracle_unpack_bits(const uint8_t* buf, int64_t n, int width, uint64_t* vals) {
    int64_t bitpos = 0;
    for (int64_t i = 0; i < n; ++i) {
        uint64_t v = 0;
        for (int b = 0; b < width; ++b) {
            v = (v << 1) | ((buf[bitpos >> 3] >> (7 - (bitpos & 7))) & 1u);
            bitpos++;
        }
        vals[i] = v;
    }
}

// Class table export (format order): per class 16 ints
// [shell, odd, w, p_req, n_word, n_free, n_vals, free_n, v0..v3(word or vals0-3), ...]
// Kept simple: callers ask for one field group at a time.
void oracle_class_range(int cap, int ci, uint64_t* lo, uint64_t* hi) {
    const Codebook& cb = book(cap);
    *lo = cb.classes[ci].offset + 1;
    *hi = cb.ends[ci];
}
void oracle_class_desc(int cap, int ci, int32_t* out /*32*/) {
    const Class& c = book(cap).classes[ci];
    std::memset(out, 0, 32 * sizeof(int32_t));
    out[0] = c.shell; out[1] = c.odd; out[2] = c.w; out[3] = c.p_req;
    if (c.odd) {
        out[4] = (int)c.vals.size();
        for (size_t t = 0; t < c.vals.size(); ++t) { out[8 + t] = c.vals[t].first; out[16 + t] = c.vals[t].second; }
    } else {
        out[4] = (int)c.word.size(); out[5] = (int)c.free_.size();
        for (size_t t = 0; t < c.word.size(); ++t) { out[8 + t] = c.word[t].first; out[16 + t] = c.word[t].second; }
        for (size_t t = 0; t < c.free_.size(); ++t) { out[12 + t] = c.free_[t].first; out[20 + t] = c.free_[t].second; }
        out[24] = c.off_counts.back();
    }
}

void oracle_golay_table(uint32_t* out /*4096*/) {
    std::memcpy(out, book12().golay.flat.data(), 4096 * sizeof(uint32_t));
}

int oracle_decode_index(int cap, uint64_t idx, int32_t* p) { return book(cap).decode_ref(idx, p) ? 1 : 0; }
int oracle_decode_index_fast(int cap, uint64_t idx, int32_t* p) { return book(cap).decode_fast(idx, p) ? 1 : 0; }
int oracle_encode_point(int cap, const int32_t* p, uint64_t* idx) { return book(cap).encode(p, idx); }
int oracle_leech_contains(const int32_t* p) { return book12().contains(p) ? 1 : 0; }

// Decode n packed 48-bit records (47-bit index, 1 gain bit) with the cap-12 book.
// points: n*24 int8; shell, gain: n bytes. Returns the count of out-of-range indices
// (their points are zero and their shell is 255).
int64_t oracle_decode_codes(const uint8_t* codes, int64_t n, int8_t* points, uint8_t* shell,
                            uint8_t* gain, int use_ref, int threads) {
    const Codebook& cb = book12();
    std::vector<int64_t> bad((size_t)std::max(threads, 1) + 1, 0);
    int64_t chunk = threads > 1 ? (n + threads - 1) / threads : n;
    parallel_rows(n, threads, [&](int64_t lo, int64_t hi) {
        int64_t nb = 0;
        int32_t p[DIM];
        for (int64_t b = lo; b < hi; ++b) {
            uint64_t v = read_code48(codes, (size_t)b);
            bool ok = use_ref ? cb.decode_ref(v >> 1, p) : cb.decode_fast(v >> 1, p);
            for (int i = 0; i < DIM; ++i) points[b * DIM + i] = (int8_t)p[i];
            shell[b] = ok ? (uint8_t)shell_of(p) : 255;
            gain[b] = (uint8_t)(v & 1);
            if (!ok) nb++;
        }
        bad[chunk > 0 ? (size_t)(lo / chunk) : 0] += nb;
    });
    int64_t tot = 0;
    for (int64_t v : bad) tot += v;
    return tot;
}

// Dense weights exactly as decode_matrix builds them (f64 arithmetic, one final
// narrowing to f32). out: d_out * d_in floats. No rotation (seed absent).
int oracle_decode_matrix(const uint8_t* codes, int d_out, int d_in, const double* centroids,
                         const double* row_scales, const float* tail, float* out, int threads) {
    const Codebook& cb = book12();
    int nb = d_in / DIM, tw = d_in % DIM;
    std::vector<int> err((size_t)1, 0);
    parallel_rows(d_out, threads, [&](int64_t lo, int64_t hi) {
        int32_t p[DIM];
        for (int64_t r = lo; r < hi; ++r) {
            for (int b = 0; b < nb; ++b) {
                uint64_t v = read_code48(codes, (size_t)(r * nb + b));
                if (!cb.decode_fast(v >> 1, p)) err[0] = 1;
                int m = shell_of(p);
                float* o = out + r * (int64_t)d_in + b * DIM;
                if (m > 0) {
                    double picked = centroids[v & 1] * row_scales[r];
                    double scale = picked / std::sqrt((double)(16 * m));
                    for (int i = 0; i < DIM; ++i) o[i] = (float)((double)p[i] * scale);
                } else {
                    for (int i = 0; i < DIM; ++i) o[i] = 0.0f;
                }
            }
            for (int t = 0; t < tw; ++t)
                out[r * (int64_t)d_in + nb * DIM + t] = (float)(double)tail[r * tw + t];
        }
    });
    return err[0];
}

// y = decode(W) * x in f64 (weights kept in f64, as matvec.rs:284-316 builds its
// reference rows), batch of nx activation vectors (row-major [nx, d_in]).
// y: [nx, d_out] f64; absdot (optional): [nx, d_out] sum |w_i x_i| for the
// reference's error criterion (matvec.rs:114-120).
int oracle_gemv_f64(const uint8_t* codes, int d_out, int d_in, const double* centroids,
                    const double* row_scales, const float* tail, const double* x, int nx,
                    double* y, double* absdot, int use_ref, int threads) {
    const Codebook& cb = book12();
    int nb = d_in / DIM, tw = d_in % DIM;
    std::vector<int> err((size_t)1, 0);
    parallel_rows(d_out, threads, [&](int64_t lo, int64_t hi) {
        int32_t p[DIM];
        std::vector<double> acc((size_t)nx), aacc((size_t)nx);
        for (int64_t r = lo; r < hi; ++r) {
            std::fill(acc.begin(), acc.end(), 0.0);
            std::fill(aacc.begin(), aacc.end(), 0.0);
            for (int b = 0; b < nb; ++b) {
                uint64_t v = read_code48(codes, (size_t)(r * nb + b));
                bool ok = use_ref ? cb.decode_ref(v >> 1, p) : cb.decode_fast(v >> 1, p);
                if (!ok) err[0] = 1;
                int m = shell_of(p);
                if (m <= 0) continue;
                double picked = centroids[v & 1] * row_scales[r];
                double scale = picked / std::sqrt((double)(16 * m));
                for (int q = 0; q < nx; ++q) {
                    const double* xb = x + (int64_t)q * d_in + b * DIM;
                    double s = 0, a = 0;
                    for (int i = 0; i < DIM; ++i) {
                        double wv = (double)p[i] * scale;
                        s += wv * xb[i];
                        a += std::fabs(wv * xb[i]);
                    }
                    acc[q] += s;
                    aacc[q] += a;
                }
            }
            for (int q = 0; q < nx; ++q) {
                const double* xt = x + (int64_t)q * d_in + nb * DIM;
                for (int t = 0; t < tw; ++t) {
                    double wv = (double)tail[r * tw + t];
                    acc[q] += wv * xt[t];
                    aacc[q] += std::fabs(wv * xt[t]);
                }
                y[(int64_t)q * d_out + r] = acc[q];
                if (absdot) absdot[(int64_t)q * d_out + r] = aacc[q];
            }
        }
    });
    return err[0];
}

int oracle_hw_threads(void) {
    unsigned n = std::thread::hardware_concurrency();
    return n ? (int)n : 1;
}

}  // extern "C"
