#include "tab_tables.h"

#include <cmath>
#include <cstring>
#include <map>

namespace llvq {

namespace {

unsigned int tab_float_bits(float f) {
    unsigned int u;
    std::memcpy(&u, &f, 4);
    return u;
}

// n! / prod c_j! as a product of binomials, exact at every step; 0 when it does not fit 32 bits
// (such states are never reached from a cap-12 class, whose arrangement counts stay below 2^31).
unsigned int multinomial_k(const int* cnt, int k) {
    unsigned __int128 total = 1;
    int placed = 0;
    for (int j = 0; j < k; ++j) {
        for (int t = 1; t <= cnt[j]; ++t) total = total * (unsigned)(placed + t) / (unsigned)t;
        placed += cnt[j];
        if (total >> 64) return 0;
    }
    return total >> 32 ? 0u : (unsigned int)total;
}

// Lexicographic unranking of one arrangement (kinds ordered by index): the plain form of
// llvq-search/src/index.rs:101-118 with the M * c / n recurrence.
void tab_unrank_arrangement(uint64_t rank, const int* cnt_in, int k, int slots, uint64_t total, int* out) {
    int cnt[8];
    for (int j = 0; j < k; ++j) cnt[j] = cnt_in[j];
    uint64_t m = total;
    for (int s = 0, n = slots; s < slots; ++s, --n) {
        for (int j = 0; j < k; ++j) {
            if (!cnt[j]) continue;
            const uint64_t mj = m * (uint64_t)cnt[j] / (uint64_t)n;
            if (rank < mj) {
                out[s] = j;
                cnt[j]--;
                m = mj;
                break;
            }
            rank -= mj;
        }
    }
}

struct Blob {
    std::vector<unsigned char>& b;
    unsigned int section(size_t bytes) {
        const size_t at = (b.size() + 15) & ~(size_t)15;
        b.resize(at + bytes, 0);
        return (unsigned int)at;
    }
    template <typename T>
    T* at(unsigned int off) {
        return reinterpret_cast<T*>(b.data() + off);
    }
};

}  // namespace

void build_tab_tables(const Codebook& cb, TabTablesHost& out) {
    out.blob.clear();
    out.lut_off.clear();
    Blob B{out.blob};
    TabLayout& L = out.layout;
    const int ncls = cb.n_classes12;

    // ---- classification: accelerator, class ends, records ----
    // Everything is keyed by the 48-bit record v = 2 idx + gain itself: class c holds the records
    // [2 (offset_c + 1), 2 (offset_c + card_c + 1)); v < 2 is the origin, v >= 2 (N12 + 1) is outside the ball.
    // lut[v >> 36] = first class whose end exceeds (v >> 36) << 36. The family of a class rides in the top
    // two bits of its first-record entry (filled in below), so classification reads nothing else.
    L.lut = B.section(4096 * 2);
    L.bounds = B.section((size_t)(ncls + 2) * 8);
    {
        uint64_t* bounds = B.at<uint64_t>(L.bounds);
        bounds[0] = 2;
        for (int c = 0; c < ncls; ++c) bounds[c + 1] = 2 * (cb.ends[c] + 1);
        bounds[ncls + 1] = 1ull << 48;
        uint16_t* lut = B.at<uint16_t>(L.lut);
        int c = 0;
        for (uint64_t b = 0; b < 4096; ++b) {
            while (c < ncls && bounds[c + 1] <= (b << 36)) ++c;
            lut[b] = (uint16_t)c;
        }
    }
    L.classify_bytes = (unsigned int)((out.blob.size() + 15) & ~(size_t)15);

    // ---- decode tables ----
    L.golay = B.section(4096 * 4);
    std::memcpy(B.at<uint32_t>(L.golay), cb.golay, 4096 * 4);
    L.spread = B.section(256 * 4);
    for (unsigned int v = 0; v < 256; ++v) {
        unsigned int e = 0;
        for (int i = 0; i < 8; ++i) e |= ((v >> i) & 1u) << (4 * i);
        B.at<uint32_t>(L.spread)[v] = e;
    }

    // three-kind state table and its tails
    L.t3 = B.section((size_t)kT3D0 * kT3D1 * kT3D2 * 8);
    L.tail3 = B.section(729 * 4);
    {
        unsigned int next = 0;
        for (int c0 = 0; c0 < kT3D0; ++c0)
            for (int c1 = 0; c1 < kT3D1; ++c1)
                for (int c2 = 0; c2 < kT3D2; ++c2) {
                    const int n = c0 + c1 + c2;
                    unsigned int* e = B.at<uint32_t>(L.t3) + 2 * ((size_t)(c0 * kT3D1 + c1) * kT3D2 + c2);
                    if (n > kDim) continue;
                    if (n == kTailSlots) {
                        const int cnt[3] = {c0, c1, c2};
                        const unsigned int m = multinomial_k(cnt, 3);
                        e[0] = next;
                        for (unsigned int r = 0; r < m; ++r) {
                            int kinds[kTailSlots];
                            tab_unrank_arrangement(r, cnt, 3, kTailSlots, m, kinds);
                            unsigned int v = 0;
                            for (int s = 0; s < kTailSlots; ++s) v |= (unsigned int)kinds[s] << (4 * s);
                            B.at<uint32_t>(L.tail3)[next++] = v;
                        }
                        continue;
                    }
                    unsigned int t0 = 0, q1 = 0;
                    if (c0 > 0) {
                        const int cnt[3] = {c0 - 1, c1, c2};
                        t0 = multinomial_k(cnt, 3);
                    }
                    if (c1 > 0) {
                        const int cnt[3] = {c0, c1 - 1, c2};
                        q1 = multinomial_k(cnt, 3);
                    }
                    e[0] = t0;
                    e[1] = t0 + q1;
                }
    }
    // four-kind tails
    L.tail4 = B.section(4096 * 4);
    L.base4 = B.section(343 * 2);
    {
        unsigned int next = 0;
        for (int c0 = 0; c0 <= kTailSlots; ++c0)
            for (int c1 = 0; c0 + c1 <= kTailSlots; ++c1)
                for (int c2 = 0; c0 + c1 + c2 <= kTailSlots; ++c2) {
                    const int cnt[4] = {c0, c1, c2, kTailSlots - c0 - c1 - c2};
                    const unsigned int m = multinomial_k(cnt, 4);
                    B.at<uint16_t>(L.base4)[c0 + 7 * (c0 + c1) + 49 * (c0 + c1 + c2)] = (uint16_t)next;
                    for (unsigned int r = 0; r < m; ++r) {
                        int kinds[kTailSlots];
                        tab_unrank_arrangement(r, cnt, 4, kTailSlots, m, kinds);
                        unsigned int v = 0;
                        for (int s = 0; s < kTailSlots; ++s) v |= (unsigned int)kinds[s] << (4 * s);
                        B.at<uint32_t>(L.tail4)[next++] = v;
                    }
                }
    }

    // ---- class records, arrangement tables of the even coset ----
    std::vector<uint16_t> lut_on;
    std::map<std::vector<int>, unsigned int> on_base, off_base, on3_base;
    std::vector<TabClass> recs((size_t)ncls);
    std::vector<unsigned int> fams((size_t)ncls, 0u);
    out.lut_on3.clear();
    out.slow_mass = 0.0;
    for (int f = 0; f < 4; ++f) out.family_mass[f] = 0.0;
    auto state3 = [](const int* cnt) { return (unsigned int)(((cnt[0] * kT3D1 + cnt[1]) * kT3D2 + cnt[2]) * 8); };
    auto fits3 = [](const int* cnt) { return cnt[0] < kT3D0 && cnt[1] < kT3D1 && cnt[2] < kT3D2; };
    for (int ci = 0; ci < ncls; ++ci) {
        const ClassInfo& c = cb.classes[ci];
        TabClass& r = recs[ci];
        std::memset(&r, 0, sizeof r);
        unsigned int fam = kFamRare, rare = kRareNone;
        r.w[0] = 0;
        r.w[1] = 0;
        r.w[3] = tab_float_bits((float)(1.0 / std::sqrt(16.0 * c.shell)));
        r.w[14] = (unsigned int)c.shell;
        if (c.odd) {
            r.w[2] = (unsigned int)c.arr_a;
            r.w[4] = tab_float_bits((float)(1.0 / (double)c.arr_a));
            int cnt[5] = {0, 0, 0, 0, 0}, val[5] = {0, 0, 0, 0, 0};
            bool served = false;
            if (c.n_a == 2 || c.n_a == 3) {
                const int shift = 3 - c.n_a;  // two-kind classes sit at c0 = 0
                for (int j = 0; j < c.n_a; ++j) {
                    cnt[j + shift] = c.cnt_a[j];
                    val[j + shift] = c.val_a[j];
                }
                if (fits3(cnt) && c.arr_a < (1ull << 31)) {
                    fam = kFamOdd3;
                    served = true;
                    r.w[5] = state3(cnt);
                }
            } else if ((c.n_a == 4 || c.n_a == 5) && c.arr_a < (1ull << 31)) {
                served = true;
                for (int j = 0; j < c.n_a; ++j) {
                    cnt[j] = c.cnt_a[j];
                    val[j] = c.val_a[j];
                }
                r.w[5] = (unsigned int)cnt[0] | (unsigned int)(cnt[0] + cnt[1]) << 8 |
                         (unsigned int)(cnt[0] + cnt[1] + cnt[2]) << 16 |
                         (unsigned int)(c.n_a == 5 ? cnt[0] + cnt[1] + cnt[2] + cnt[3] : 0) << 24;
                if (c.n_a == 4) fam = kFamOdd4; else rare = kRareOdd5;
            }
            if (served) {
                // forced signs (index.rs:424-430): a value = 3 (mod 4) is positive on the codeword
                // support and negative off it; a value = 1 (mod 4) the opposite.
                unsigned int lo = 0, hi = 0;
                int on[5];
                for (int j = 0; j < 5; ++j) on[j] = (val[j] & 3) == 3 ? val[j] : -val[j];
                for (int j = 0; j < 4; ++j) {
                    hi |= (unsigned int)(uint8_t)(int8_t)on[j] << (8 * j);
                    lo |= (unsigned int)(uint8_t)(int8_t)(-on[j]) << (8 * j);
                }
                if (rare == kRareOdd5) {
                    r.w[6] = hi;  // on-support values of kinds 0-3
                    r.w[7] = (unsigned int)(uint8_t)(int8_t)on[4];
                } else {
                    r.w[6] = lo;
                    r.w[7] = hi;
                }
            }
        } else if (c.w == 24 && c.n_a >= 1 && c.n_a <= 3 && c.n_b == 1) {
            // every position on the support: the on-support arrangement is a 24-slot problem
            int cnt[3] = {0, 0, 0}, val[3] = {0, 0, 0};
            const int shift = 3 - c.n_a;
            for (int j = 0; j < c.n_a; ++j) {
                cnt[j + shift] = c.cnt_a[j];
                val[j + shift] = c.val_a[j];
            }
            if (fits3(cnt)) {
                rare = kRareW24;
                r.w[4] = (unsigned int)c.p_req;
                r.w[5] = state3(cnt);
                for (int j = 0; j < 3; ++j) {
                    r.w[6] |= (unsigned int)(uint8_t)val[j] << (8 * j);
                    r.w[7] |= (unsigned int)(uint8_t)(int8_t)(-val[j]) << (8 * j);
                }
            }
        } else if (c.w == 0 && (c.n_b == 2 || c.n_b == 3) && c.val_b[c.n_b - 1] == 0) {
            // empty support: the off-support arrangement is a 24-slot problem whose last kind is the zero run
            int cnt[3] = {0, 0, 0}, val[3] = {0, 0, 0};
            const int shift = 3 - c.n_b;
            for (int j = 0; j < c.n_b; ++j) {
                cnt[j + shift] = c.cnt_b[j];
                val[j + shift] = c.val_b[j];
            }
            if (fits3(cnt) && c.arr_b < (1ull << 31)) {
                rare = kRareW0;
                r.w[2] = (unsigned int)c.arr_b;
                r.w[4] = (unsigned int)c.free_n;
                r.w[5] = state3(cnt);
                for (int j = 0; j < 3; ++j) {
                    r.w[6] |= (unsigned int)(uint8_t)val[j] << (8 * j);
                    r.w[7] |= (unsigned int)(uint8_t)(int8_t)(-val[j]) << (8 * j);
                }
            }
        } else {
            r.w[2] = (unsigned int)c.arr_b;
            const int slots_b = kDim - c.w;
            const bool ok = (c.w == 8 || c.w == 12 || c.w == 16) && c.n_a >= 1 && c.n_a <= 3 && c.n_b <= 4 &&
                            c.arr_b <= kOffLutCap;
            if (ok) {
                if (c.n_a == 3) rare = kRareOn3; else fam = kFamEven;
                std::vector<int> key_on = {c.w}, key_off = {slots_b};
                int cnt_a[3] = {0, 0, 0}, cnt_b[4] = {0, 0, 0, 0};
                for (int j = 0; j < c.n_a; ++j) {
                    key_on.push_back(c.cnt_a[j]);
                    cnt_a[j] = c.cnt_a[j];
                }
                for (int j = 0; j < c.n_b; ++j) {
                    key_off.push_back(c.cnt_b[j]);
                    key_off.push_back(c.val_b[j] != 0);
                    cnt_b[j] = c.cnt_b[j];
                }
                if (c.n_a == 3) {
                    if (!on3_base.count(key_on)) {
                        on3_base[key_on] = (unsigned int)out.lut_on3.size();
                        int kinds[kDim];
                        for (uint64_t rk = 0; rk < c.arr_a; ++rk) {
                            tab_unrank_arrangement(rk, cnt_a, c.n_a, c.w, c.arr_a, kinds);
                            unsigned long long e = 0;
                            for (int s = 0; s < c.w; ++s) e |= (unsigned long long)kinds[s] << (4 * s);
                            out.lut_on3.push_back(e);
                        }
                    }
                    r.w[8] = on3_base[key_on];
                } else {
                    if (!on_base.count(key_on)) {
                        on_base[key_on] = (unsigned int)lut_on.size();
                        int kinds[kDim];
                        for (uint64_t rk = 0; rk < c.arr_a; ++rk) {
                            tab_unrank_arrangement(rk, cnt_a, c.n_a, c.w, c.arr_a, kinds);
                            unsigned int e = 0;
                            for (int s = 0; s < c.w; ++s) e |= (unsigned int)kinds[s] << s;
                            lut_on.push_back((uint16_t)e);
                        }
                    }
                    r.w[8] = on_base[key_on];
                }
                if (!off_base.count(key_off)) {
                    off_base[key_off] = (unsigned int)out.lut_off.size();
                    int kinds[kDim];
                    for (uint64_t rk = 0; rk < c.arr_b; ++rk) {
                        tab_unrank_arrangement(rk, cnt_b, c.n_b, slots_b, c.arr_b, kinds);
                        OffEntry e{0, 0, 0, 0};
                        unsigned int nz = 0;
                        for (int s = 0; s < slots_b; ++s) {
                            (s < 8 ? e.klo : e.khi) |= (unsigned int)kinds[s] << (4 * (s & 7));
                            // the zero run is recognised by its value, never by its kind index
                            if (c.val_b[kinds[s]] != 0) nz |= 1u << s;
                        }
                        e.nz = nz | (unsigned int)__builtin_popcount(nz & 0xfu) << 16 |
                               (unsigned int)__builtin_popcount(nz & 0xffu) << 20 |
                               (unsigned int)__builtin_popcount(nz & 0xfffu) << 24;
                        out.lut_off.push_back(e);
                    }
                }
                unsigned int m_off, s_off, m_on, s_on;
                magic28((unsigned int)c.arr_b, &m_off, &s_off);
                magic28((unsigned int)c.arr_a, &m_on, &s_on);
                r.w[4] = (unsigned int)c.arr_a | (unsigned int)c.w << 16 | (unsigned int)c.free_n << 24 |
                         (unsigned int)c.p_req << 31;
                r.w[5] = m_off;
                r.w[6] = m_on;
                r.w[7] = s_off | s_on << 8 | (unsigned int)cb.bucket[c.w] << 16;
                r.w[9] = off_base[key_off];
                for (int j = 0; j < c.n_a; ++j) {
                    r.w[10] |= (unsigned int)(uint8_t)c.val_a[j] << (8 * j);
                    r.w[11] |= (unsigned int)(uint8_t)(int8_t)(-(int)c.val_a[j]) << (8 * j);
                }
                for (int j = 0; j < c.n_b; ++j) {
                    r.w[12] |= (unsigned int)(uint8_t)c.val_b[j] << (8 * j);
                    r.w[13] |= (unsigned int)(uint8_t)(int8_t)(-(int)c.val_b[j]) << (8 * j);
                }
            }
        }
        r.w[15] = rare;
        fams[ci] = fam;
        const double mass = (double)c.card / (double)cb.total12;
        out.family_mass[fam] += mass;
        if (fam == kFamRare && rare == kRareNone) out.slow_mass += mass;
    }
    for (int ci = 0; ci < ncls; ++ci) B.at<uint64_t>(L.bounds)[ci] |= (uint64_t)fams[ci] << 62;
    // the records do not belong to what classification reads: they follow the decode tables
    L.cls = B.section((size_t)ncls * kClsStride);
    for (int ci = 0; ci < ncls; ++ci) std::memcpy(out.blob.data() + L.cls + (size_t)ci * kClsStride, &recs[ci], sizeof(TabClass));

    L.lut_on = B.section(lut_on.size() * 2);
    std::memcpy(B.at<uint16_t>(L.lut_on), lut_on.data(), lut_on.size() * 2);

    L.pat = B.section(16 * 4);
    for (unsigned int c = 0; c < 16; ++c) {
        unsigned int sel = 0, ones = 0, zeros = 0;
        for (int i = 0; i < 4; ++i) {
            if ((c >> i) & 1u)
                sel |= ones++ << (4 * i);
            else
                sel |= (4u + zeros++) << (4 * i);
        }
        B.at<uint32_t>(L.pat)[c] = sel | ones << 16;
    }
    L.pd4 = B.section(256 * 2);
    for (unsigned int v = 0; v < 256; ++v) {
        const unsigned int nz = v & 15u;
        unsigned int sf = v >> 4, e = 0;
        for (int i = 0; i < 4; ++i)
            if ((nz >> i) & 1u) {
                e |= (sf & 1u) << (4 * i + 2);
                sf >>= 1;
            }
        B.at<uint16_t>(L.pd4)[v] = (uint16_t)e;
    }
    L.total_bytes = (unsigned int)((out.blob.size() + 15) & ~(size_t)15);
    out.blob.resize(L.total_bytes, 0);
}

}  // namespace llvq
